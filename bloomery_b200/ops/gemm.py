"""Python face of the tcgen05 grouped GEMM (``csrc/gemm_tcgen05.cu``) and its helpers
(``csrc/prefill_aux.cu``)."""
from __future__ import annotations

from typing import Optional

import torch

from ._lib import F, I, L, check, cuda, p, stream
from .decode import QWeight, sm_count

BM = 128


class TileTable:
    """Device-resident table of row tiles of a (grouped) GEMM: 128 rows per tile, or ``tile_rows`` for the
    quantised-weight GEMM, whose token tiles may be 32 rows."""

    def __init__(self, max_rows: int, n_groups: int, device, tile_rows: int = BM):
        self.tile_rows = tile_rows
        self.max_mtiles = max_rows // tile_rows + n_groups + 1
        self.n_groups = n_groups
        self.mtiles = torch.zeros(self.max_mtiles, 4, dtype=torch.int32, device=device)
        self.n_mtiles = torch.zeros(1, dtype=torch.int32, device=device)
        self.offsets = torch.zeros(n_groups + 1, dtype=torch.int32, device=device)

    def build(self, group_rows: torch.Tensor, group_div: int = 1, group_stride: int = 0, base: int = 0,
              causal_pos0: int = -1, causal_kind: int = 0) -> None:
        """group_rows int32 [n_groups] on the device.  Rows of group g follow group g-1 in A
        (or start at ``base + g * group_stride`` when ``group_stride`` > 0) and use B matrix
        ``g // group_div``."""
        if causal_kind:
            # causal_kind 1: the product's columns are keys (scores), 2: its depth is keys (values); row r of a group
            # is the query at position causal_pos0 + r: tiles beyond the diagonal are skipped / cut short
            check(cuda().bl_gemm_build_tiles_causal(p(group_rows), I(self.n_groups), p(self.mtiles), p(self.n_mtiles),
                                                    I(self.max_mtiles), p(self.offsets), I(group_div), I(group_stride),
                                                    I(base), I(causal_pos0), I(causal_kind), stream()),
                  "bl_gemm_build_tiles_causal")
            return
        check(cuda().bl_gemm_build_tiles(p(group_rows), I(self.n_groups), p(self.mtiles), p(self.n_mtiles),
                                         I(self.max_mtiles), p(self.offsets), I(group_div), I(group_stride), I(base),
                                         stream()), "bl_gemm_build_tiles")

    @classmethod
    def sharded(cls, total_rows: int, src_rows: int, device) -> "TileTable":
        """Dense product whose A rows live on several ranks in blocks of ``src_rows`` (a multiple of 128)."""
        t = cls(total_rows, total_rows // src_rows + 1, device)
        check(cuda().bl_gemm_build_tiles_sharded(p(torch.tensor([total_rows], dtype=torch.int32, device=device)),
                                                 p(t.mtiles), p(t.n_mtiles), I(t.max_mtiles), I(src_rows), stream()),
              "bl_gemm_build_tiles_sharded")
        return t

    @classmethod
    def dense(cls, rows: int, device, tile_rows: int = BM) -> "TileTable":
        t = cls(rows, 1, device, tile_rows)
        if tile_rows == BM:
            t.build(torch.tensor([rows], dtype=torch.int32, device=device))
        else:
            rows0 = list(range(0, rows, tile_rows))
            t.mtiles[:len(rows0)] = torch.tensor([[0, r, rows, 0] for r in rows0], dtype=torch.int32).to(device)
            t.n_mtiles.fill_(len(rows0))
            t.offsets.copy_(torch.tensor([0, rows], dtype=torch.int32))
        return t


def gemm_bf16(A: torch.Tensor, B: torch.Tensor, tiles: TileTable, *, out_f32: Optional[torch.Tensor] = None,
              out_bf16: Optional[torch.Tensor] = None, B2: Optional[torch.Tensor] = None, dst_row=None, row_scale=None,
              resid=None, status: Optional[torch.Tensor] = None) -> None:
    """C = A @ B[g].T per tile.  A [rows, K] bf16; B (and B2) [G, N, K] or [N, K] bf16.
    With B2 the output is silu(A B^T) * (A B2^T)."""
    assert A.dtype == torch.bfloat16 and B.dtype == torch.bfloat16 and A.stride(-1) == 1 and B.is_contiguous()
    if B.dim() == 2:
        B = B[None]
        B2 = B2[None] if B2 is not None else None
    G, N, Kd = B.shape
    out = out_f32 if out_f32 is not None else out_bf16
    rc = cuda().bl_gemm_bf16(p(A), L(A.stride(0)), L(A.shape[0]), p(B), p(B2), I(G), I(N), I(Kd), p(tiles.mtiles),
                             p(tiles.n_mtiles), I(tiles.max_mtiles), p(out_f32), p(out_bf16), L(out.stride(0)),
                             p(dst_row), p(row_scale), p(resid), L(resid.stride(0) if resid is not None else 0),
                             p(status), I(sm_count()), stream())
    check(rc, "bl_gemm_bf16")


def _ptr_array(ptrs):
    import ctypes
    return (ctypes.c_void_p * len(ptrs))(*[int(x) for x in ptrs])


def gemm_bf16_dist(A_ptrs, rows_a: int, lda: int, B: torch.Tensor, tiles: TileTable, *, src_rows: int = 0,
                   out_f32: Optional[torch.Tensor] = None, out_bf16: Optional[torch.Tensor] = None,
                   B2: Optional[torch.Tensor] = None, dst_row=None, row_scale=None, owners=None, rows_per_owner: int = 0,
                   ldc: int = 0, dst_div: int = 1, status: Optional[torch.Tensor] = None) -> None:
    """The several-GPU form of :func:`gemm_bf16`.  ``A_ptrs``: device addresses of every source rank's A shard
    ([rows_a, K] bf16 each; one entry = local rows only).  ``owners``: device addresses of every rank's fp32
    output shard; when given, product rows are added into the shard of the rank that owns them
    (row // rows_per_owner) instead of being stored."""
    if B.dim() == 2:
        B = B[None]
        B2 = B2[None] if B2 is not None else None
    G, N, Kd = B.shape
    out = out_f32 if out_f32 is not None else out_bf16
    rc = cuda().bl_gemm_bf16_dist(_ptr_array(A_ptrs), I(len(A_ptrs)), L(lda), L(rows_a), p(B), p(B2), I(G), I(N), I(Kd),
                                  p(tiles.mtiles), p(tiles.n_mtiles), I(tiles.max_mtiles), p(out_f32), p(out_bf16),
                                  L(out.stride(0) if out is not None else ldc), p(dst_row), p(row_scale),
                                  _ptr_array(owners) if owners else None, I(len(owners) if owners else 0),
                                  I(rows_per_owner), I(dst_div), I(src_rows), p(status), I(sm_count()), stream())
    check(rc, "bl_gemm_bf16_dist")


def rank_barrier(peer_flag_ptrs, my_flags_ptr: int, epoch: int, rank: int, status: Optional[torch.Tensor]) -> None:
    import ctypes
    check(cuda().bl_rank_barrier(_ptr_array(peer_flag_ptrs), ctypes.c_void_p(my_flags_ptr), ctypes.c_uint(epoch & 0xFFFFFFFF),
                                 I(len(peer_flag_ptrs)), I(rank), p(status), stream()), "bl_rank_barrier")


def rank_barrier_step(peer_flag_ptrs, my_flags_ptr: int, step: torch.Tensor, sites_per_step: int, site: int, rank: int,
                      status: Optional[torch.Tensor]) -> None:
    """The barrier of a captured pass: its epoch comes from the device-side pass counter ``step``."""
    import ctypes
    check(cuda().bl_rank_barrier_step(_ptr_array(peer_flag_ptrs), ctypes.c_void_p(my_flags_ptr), p(step),
                                      ctypes.c_uint(sites_per_step), ctypes.c_uint(site), I(len(peer_flag_ptrs)), I(rank),
                                      p(status), stream()), "bl_rank_barrier_step")


def push_rows(src: torch.Tensor, dst_ptrs, n_bytes: int) -> None:
    """``n_bytes`` of ``src`` into every address of ``dst_ptrs`` (peer pointers included)."""
    check(cuda().bl_push_rows(p(src), _ptr_array(dst_ptrs), I(len(dst_ptrs)), L(n_bytes), stream()), "bl_push_rows")


def sum_ranks(gathered: torch.Tensor, slot_stride: int, n_ranks: int, x: torch.Tensor, n: int) -> None:
    """x[:n] += gathered[0][:n] + gathered[1][:n] + ... in rank order (fp32; ``slot_stride`` floats between slots)."""
    check(cuda().bl_sum_ranks(p(gathered), L(slot_stride), I(n_ranks), p(x), L(n), stream()), "bl_sum_ranks")


def gather_rows_peer(src_ptrs, src_stride: int, rows_per_rank: int, dst_row, n_rows, max_rows: int, k: int, K_: int, out) -> None:
    check(cuda().bl_gather_rows_peer(_ptr_array(src_ptrs), I(len(src_ptrs)), L(src_stride), I(rows_per_rank), p(dst_row),
                                     p(n_rows), I(max_rows), I(k), I(K_), p(out), stream()), "bl_gather_rows_peer")


def copy_bytes(src_ptr: int, dst_ptr: int, n_bytes: int) -> None:
    import ctypes
    check(cuda().bl_copy_bytes(ctypes.c_void_p(src_ptr), ctypes.c_void_p(dst_ptr), L(n_bytes), stream()), "bl_copy_bytes")


def localize_ids(ids: torch.Tensor, e_lo: int, e_hi: int, out: torch.Tensor) -> None:
    check(cuda().bl_localize_ids(p(ids), I(ids.numel()), I(e_lo), I(e_hi), p(out), stream()), "bl_localize_ids")


def dequant_bf16(w: QWeight, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Expand a resident quantised weight (matrix or stack) to bf16 [..., rows, K]."""
    lead = w.data.shape[:-1]
    rows = 1
    for d in lead:
        rows *= d
    if out is None:
        out = torch.empty(*lead, w.k, dtype=torch.bfloat16, device=w.data.device)
    check(cuda().bl_dequant_bf16(p(w.data), I(w.wt), L(rows), I(w.k), p(out), stream()), "bl_dequant_bf16")
    return out


def rmsnorm_bf16(x: torch.Tensor, gain: Optional[torch.Tensor], eps: float, out: torch.Tensor) -> None:
    check(cuda().bl_rmsnorm_bf16(p(x), L(x.stride(0)), p(gain), F(eps), I(x.shape[0]), I(x.shape[1]), p(out),
                                 L(out.stride(0)), stream()), "bl_rmsnorm_bf16")


def moe_count(ids: torch.Tensor, E: int, counts: torch.Tensor) -> None:
    check(cuda().bl_moe_count(p(ids), I(ids.numel()), I(E), p(counts), stream()), "bl_moe_count")


def moe_scatter(ids, wts, E: int, offsets, cursor, pos_of, dst_row, row_scale) -> None:
    check(cuda().bl_moe_scatter(p(ids), p(wts), I(ids.numel()), I(E), p(offsets), p(cursor), p(pos_of), p(dst_row),
                                p(row_scale), stream()), "bl_moe_scatter")


def gather_rows_bf16(src, dst_row, n_rows, max_rows: int, k: int, out) -> None:
    check(cuda().bl_gather_rows_bf16(p(src), L(src.stride(0)), p(dst_row), p(n_rows), I(max_rows), I(k),
                                     I(src.shape[1]), p(out), stream()), "bl_gather_rows_bf16")


def moe_combine(slot_out, pos_of, T: int, k: int, resid, out) -> None:
    check(cuda().bl_moe_combine(p(slot_out), p(pos_of), I(T), I(k), I(out.shape[1]), p(resid),
                                L(resid.stride(0) if resid is not None else 0), p(out), L(out.stride(0)), stream()),
          "bl_moe_combine")


def kv_gather_bf16(k_cache, v_cache, block_table_row, n_pages: int, n_kv: int, head: int, n_keys: int, T_pad: int, Kb, Vt):
    check(cuda().bl_kv_gather_bf16(p(k_cache), p(v_cache), p(block_table_row), I(n_pages), I(n_kv), I(head), I(n_keys),
                                   I(T_pad), p(Kb), p(Vt), stream()), "bl_kv_gather_bf16")


def flash_prefill(q_bf: torch.Tensor, Kb: torch.Tensor, Vt: torch.Tensor, out: torch.Tensor, pos0: int,
                  status: Optional[torch.Tensor] = None) -> None:
    """Causal attention of a prompt chunk on tcgen05 tiles (``csrc/flash_tcgen05.cu``): queries bf16 [n_q, T, 128]
    (normalised, rotated, pre-scaled) at positions pos0.., keys bf16 [n_kv, T_pad, 128], values transposed bf16
    [n_kv, 128, T_pad] (columns past the last key zero), output bf16 [T, n_q * 128]."""
    n_q, T, hd = q_bf.shape
    n_kv, T_pad, _ = Kb.shape
    assert hd == 128 and Vt.shape == (n_kv, 128, T_pad) and q_bf.is_contiguous() and Kb.is_contiguous() and Vt.is_contiguous()
    rc = cuda().bl_flash_prefill(p(q_bf), p(Kb), p(Vt), p(out), L(out.stride(0)), I(T), I(n_q), I(n_kv), I(pos0), I(T_pad),
                                 p(status), stream())
    check(rc, "bl_flash_prefill")


def softmax_causal(S, rows: int, Tq: int, pos0: int, T_pad: int, P) -> None:
    check(cuda().bl_softmax_causal(p(S), L(S.stride(0)), L(rows), I(Tq), I(pos0), I(T_pad), p(P), L(P.stride(0)),
                                   stream()), "bl_softmax_causal")


def moe_plan(ids, wts, E: int, tiles: "TileTable", pos_of, dst_row, row_scale) -> None:
    """Count, offsets, tile table and scatter of a micro-batch's routed slots in one launch (``ids`` / ``wts`` flat)."""
    n = ids.numel()
    rc = cuda().bl_moe_plan(p(ids), p(wts), I(n), I(E), I(dst_row.numel()), p(tiles.offsets), p(pos_of), p(dst_row),
                            p(row_scale), p(tiles.mtiles), p(tiles.n_mtiles), I(tiles.max_mtiles), I(tiles.tile_rows),
                            stream())
    check(rc, "bl_moe_plan")


def qgemm_supports(w: QWeight) -> bool:
    return bool(cuda().bl_qgemm_supports(I(w.wt))) and w.k % 256 == 0


def qgemm(X: torch.Tensor, W: QWeight, tiles: TileTable, *, out_f32: Optional[torch.Tensor] = None,
          out_bf16: Optional[torch.Tensor] = None, W2: Optional[QWeight] = None, dst_row=None, row_scale=None,
          resid=None, status: Optional[torch.Tensor] = None) -> None:
    """C = X @ W[g].T per token tile with W left block-quantised (``csrc/qgemm_tcgen05.cu``): X [rows, K] bf16, W (and
    W2) resident Q4_K / Q5_K / Q6_K / Q8_0 / FP8_B128 / NVFP4 / Q8_F32 matrices [N, bytes] or stacks [G, N, bytes]; tiles of
    32, 64 or 128 token rows.
    With W2 the output is silu(X W^T) * (X W2^T)."""
    assert X.dtype == torch.bfloat16 and X.stride(-1) == 1 and W.data.is_contiguous() and tiles.tile_rows in (32, 64, 128)
    assert W2 is None or (W2.wt == W.wt and W2.data.shape == W.data.shape and W2.data.is_contiguous())
    G = W.data.shape[0] if W.data.dim() == 3 else 1
    N = W.data.shape[-2]
    out = out_f32 if out_f32 is not None else out_bf16
    rc = cuda().bl_qgemm(p(X), L(X.stride(0)), L(X.shape[0]), p(W.data), p(W2.data if W2 is not None else None), I(W.wt),
                         I(G), I(N), I(W.k), p(tiles.mtiles), p(tiles.n_mtiles), I(tiles.max_mtiles), I(tiles.tile_rows),
                         p(out_f32), p(out_bf16), L(out.stride(0)), p(dst_row), p(row_scale), p(resid),
                         L(resid.stride(0) if resid is not None else 0), p(status), I(sm_count()), stream())
    check(rc, "bl_qgemm")


def fp8_rows(x: torch.Tensor, codes: torch.Tensor, scales: torch.Tensor, gain: Optional[torch.Tensor] = None,
             eps: float = 0.0) -> None:
    """E4M3 codes [M, K] (uint8) and 1 x 128 scales [M, K / 128] of the rows of ``x`` (bf16, or fp32 with an RMSNorm of
    gain ``gain`` applied first): the activation side of :func:`fp8_gemm`."""
    assert x.stride(-1) == 1 and codes.dtype == torch.uint8 and codes.stride(-1) == 1 and scales.is_contiguous()
    assert x.dtype in (torch.bfloat16, torch.float32) and (gain is None or x.dtype == torch.float32)
    M, Kd = x.shape
    assert scales.shape[-1] == Kd // 128 and codes.shape[-1] == Kd
    check(cuda().bl_fp8_rows(p(x), I(1 if x.dtype == torch.float32 else 0), L(x.stride(0)), p(gain), F(eps), I(M), I(Kd),
                             p(codes), L(codes.stride(0)), p(scales), stream()), "bl_fp8_rows")


def fp8_gemm(Xq: torch.Tensor, xs: torch.Tensor, W: QWeight, tiles: TileTable, *, out_f32: Optional[torch.Tensor] = None,
             out_bf16: Optional[torch.Tensor] = None, W2: Optional[QWeight] = None, dst_row=None, row_scale=None,
             resid=None, status: Optional[torch.Tensor] = None) -> None:
    """The block-scaled FP8 product (``csrc/fp8gemm_tcgen05.cu``): both operands E4M3 into tcgen05 ``kind::f8f6f4``, the
    128-wide partial sums promoted to fp32 with the weight block's and the activation row's scale.  ``Xq`` / ``xs``:
    :func:`fp8_rows`; W (and W2) resident FP8_B128 matrices or stacks; tiles of 32 token rows.  Same epilogue options
    as :func:`qgemm`."""
    assert Xq.dtype == torch.uint8 and Xq.stride(-1) == 1 and xs.is_contiguous() and W.qtype == "FP8_B128"
    assert W.data.is_contiguous() and tiles.tile_rows == 32 and Xq.shape[-1] == W.k and xs.shape == (Xq.shape[0], W.k // 128)
    assert W2 is None or (W2.wt == W.wt and W2.data.shape == W.data.shape and W2.data.is_contiguous())
    G = W.data.shape[0] if W.data.dim() == 3 else 1
    N = W.data.shape[-2]
    out = out_f32 if out_f32 is not None else out_bf16
    rc = cuda().bl_fp8_gemm(p(Xq), L(Xq.stride(0)), L(Xq.shape[0]), p(xs), p(W.data), p(W2.data if W2 is not None else None),
                            I(G), I(N), I(W.k), p(tiles.mtiles), p(tiles.n_mtiles), I(tiles.max_mtiles), I(tiles.tile_rows),
                            p(out_f32), p(out_bf16), L(out.stride(0)), p(dst_row), p(row_scale), p(resid),
                            L(resid.stride(0) if resid is not None else 0), p(status), I(sm_count()), stream())
    check(rc, "bl_fp8_gemm")


def qk_norm_rope_append_prefill(qkv, q_gain, k_gain, inv_freq, eps, q_scale, head, n_q, n_kv, T, row_pos, row_seq,
                                block_table, n_pages, k_cache, v_cache, q_bf16, fault, layer) -> None:
    """Per-head RMSNorm + RoPE + KV append of T prompt rows: a block per token, a warp per head."""
    rc = cuda().bl_rope_append_prefill(p(qkv), L(qkv.stride(0)), p(q_gain), p(k_gain), p(inv_freq), F(eps),
                                       F(q_scale), I(head), I(n_q), I(n_kv), I(T), p(row_pos), p(row_seq),
                                       p(block_table), I(block_table.shape[1]), I(n_pages), p(k_cache),
                                       p(v_cache), p(q_bf16), p(fault), I(layer), stream())
    check(rc, "bl_rope_append_prefill")


def rmsnorm_hilo(x: torch.Tensor, gain: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """out [T, 3K] bf16 = [hi | hi | lo] of RMSNorm(x) * gain (split-precision router rows)."""
    check(cuda().bl_rmsnorm_hilo(p(x), L(x.stride(0)), p(gain), F(eps), I(x.shape[0]), I(x.shape[1]), p(out), stream()),
          "bl_rmsnorm_hilo")


def hilo_weights(w_f32: torch.Tensor) -> torch.Tensor:
    """[E, K] fp32 -> [E, 3K] bf16 = [Whi | Wlo | Whi], the partner of :func:`rmsnorm_hilo`."""
    hi = w_f32.bfloat16()
    lo = (w_f32 - hi.float()).bfloat16()
    return torch.cat([hi, lo, hi], 1).contiguous()
