"""Launch contracts of the CUDA library, exercised without a card: every entry point checks shapes, types, alignment and
limits before it touches the device and answers a negative code (``BL_ERR_SHAPE`` -2, ``BL_ERR_TYPE`` -3,
``BL_ERR_ALIGN`` -4, ``BL_ERR_LIMIT`` -5) that ``bl_error_string`` names.  The pointers below are never dereferenced:
each call is refused first.  (The reference keeps the same kind of suite for its device contract,
``crates/device/src/fault.rs`` and the launch checks of ``crates/chain``.)"""
import ctypes

import pytest

from bloomery_b200.ops._lib import KernelError, check, cuda

SHAPE, TYPE, ALIGN, LIMIT = -2, -3, -4, -5
I, L, F, P = ctypes.c_int, ctypes.c_long, ctypes.c_float, ctypes.c_void_p
A = 0x10000          # an aligned address nothing reads
WT_Q4_K, WT_F32, WT_FP8_B128 = 12, 0, 41


def _qgemm(K=1024, N=256, wtype=WT_Q4_K, tile_rows=32, x=A, ldx=None, c_f32=A, c_bf16=0, rows=64):
    return cuda().bl_qgemm(P(x), L(K if ldx is None else ldx), L(rows), P(A), P(0), I(wtype), I(1), I(N), I(K), P(A), P(A), I(4),
                           I(tile_rows), P(c_f32), P(c_bf16), L(N), P(0), P(0), P(0), L(0), P(0), I(148), P(0))


def test_quantised_gemm_refuses_before_it_launches():
    assert _qgemm(K=1000) == SHAPE                    # K not a multiple of 256
    assert _qgemm(tile_rows=48) == SHAPE
    assert _qgemm(c_f32=A, c_bf16=A) == SHAPE         # exactly one output
    assert _qgemm(c_f32=0, c_bf16=0) == SHAPE
    assert _qgemm(x=A + 2) == ALIGN
    assert _qgemm(ldx=1028) == ALIGN                  # rows of X not 16-byte multiples
    assert _qgemm(wtype=WT_F32) == TYPE               # float rows have no expander
    assert _qgemm(wtype=99) == TYPE
    assert cuda().bl_qgemm_supports(I(WT_Q4_K)) == 1 and cuda().bl_qgemm_supports(I(WT_FP8_B128)) == 1
    assert cuda().bl_qgemm_supports(I(WT_F32)) == 0


def _fp8_gemm(K=1024, tile_rows=32, x=A, ldx=None, c_f32=A, c_bf16=0):
    return cuda().bl_fp8_gemm(P(x), L(K if ldx is None else ldx), L(64), P(A), P(A), P(0), I(1), I(256), I(K), P(A), P(A), I(4),
                              I(tile_rows), P(c_f32), P(c_bf16), L(256), P(0), P(0), P(0), L(0), P(0), I(148), P(0))


def test_block_scaled_fp8_entries_refuse_before_they_launch():
    assert _fp8_gemm(K=1000) == SHAPE
    assert _fp8_gemm(tile_rows=64) == SHAPE           # this kernel takes 32-token tiles only
    assert _fp8_gemm(c_f32=A, c_bf16=A) == SHAPE
    assert _fp8_gemm(x=A + 4) == ALIGN
    assert _fp8_gemm(ldx=1000) == ALIGN
    rows = lambda **kw: cuda().bl_fp8_rows(P(kw.get("x", A)), I(kw.get("f32", 0)), L(kw.get("ldx", 1024)), P(kw.get("gain", 0)), F(1e-6),  # noqa: E731
                                           I(kw.get("M", 4)), I(kw.get("K", 1024)), P(A), L(kw.get("ldc", 1024)), P(A), P(0))
    assert rows(K=1000) == SHAPE and rows(M=0) == SHAPE and rows(ldc=1000) == SHAPE
    assert rows(x=A + 8) == ALIGN
    assert rows(gain=A, f32=0) == TYPE                # the fused norm reads fp32 rows


def test_attention_and_router_entries_refuse_before_they_launch():
    lib = cuda()
    kv = lambda lora, rope, M: lib.bl_mla_kv_append(P(A), L(576), P(A), P(A), F(1e-6), I(lora), I(rope), I(M), P(A), P(A), P(A),  # noqa: E731
                                                    I(4), I(16), P(A), P(A), I(0), P(0))
    assert kv(256, 64, 1) == SHAPE and kv(512, 32, 1) == SHAPE and kv(512, 64, 0) == SHAPE
    router = lambda E, K, M, wt: lib.bl_router(P(A), L(K), P(A), F(1e-6), P(A), I(wt), I(K), I(E), I(M), P(A), P(0), P(0), P(0),  # noqa: E731
                                               P(0), P(A), I(0), P(0), P(0), I(8), I(0), I(1), F(1.0), I(1), I(1), P(0), P(0), P(0),
                                               P(0), P(0), P(0), L(0), L(0), P(0), P(0))
    assert router(100000, 2048, 1, WT_F32) == LIMIT   # more experts than the routing block holds
    assert router(128, 1000, 1, WT_F32) == SHAPE
    assert router(128, 2048, 1, WT_Q4_K) == TYPE      # router weights are float rows


def test_every_code_has_a_name_and_check_raises_it():
    names = {code: cuda().bl_error_string(I(code)).decode() for code in (SHAPE, TYPE, ALIGN, LIMIT)}
    assert len(set(names.values())) == 4 and all(names.values())
    with pytest.raises(KernelError, match=r"bl_qgemm: .* \(code -2\)"):
        check(_qgemm(K=1000), "bl_qgemm")
    check(0, "nothing")
